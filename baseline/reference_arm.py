"""The reference arm of ``bench.py``: nesmind/matricxon's own code, unmodified, on the same
metric and configuration.

Nothing of this repository's engine, models or kernels runs here. The reference tree is
expected under ``baseline/_ref`` (``app/`` and ``tools/``); pip cannot install it (it has no
package metadata), so it is a plain copy put on ``sys.path``, the way the reference's own
tests find it (pyproject.toml: ``pythonpath = ["."]``).

What runs, all of it the reference's stock path:
  * the random StarCoder2 weights are written as a BF16 GGUF with the reference's
    ``GGUFBuilder`` (tools/make_tiny_gguf.py:24-116) and read back by ``GGUFModelLoader``
    (app/gguf/loader.py:12-50) into ``Starcoder2Architecture.from_gguf``
    (app/architectures/starcoder2.py:112-127), placed on the GPU by ``place_on``
    (app/architectures/device_placement.py:27-61) with the dtype ``ComputeDevice.load_dtype``
    picks (app/runtime/compute_device.py:74-79);
  * every request is a ``ChatEngine.stream_steps`` coroutine (app/runtime/chat_engine.py:109-205):
    it prefills its prompt in the reference's 256-token pieces and then asks for one
    ``DecodeStep`` per token; the pending steps of all requests go to ``BatchDecoder.decode``
    (app/runtime/batch_decode.py:63-87) in one call, as the reference's worker does
    (app/models/worker.py:177-179), and each coroutine samples its token on the host.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REFERENCE_ROOT = HERE / "_ref"


class ReferenceUnavailable(RuntimeError):
    pass


def import_reference():
    if not (REFERENCE_ROOT / "app" / "architectures" / "starcoder2.py").is_file():
        raise ReferenceUnavailable(
            f"no copy of nesmind/matricxon under {REFERENCE_ROOT} (pip cannot install it: the tree has "
            "no package metadata; a plain copy of its app/ and tools/ folders is expected there)")
    if str(REFERENCE_ROOT) not in sys.path:
        sys.path.insert(0, str(REFERENCE_ROOT))
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    sys.dont_write_bytecode = True


def write_random_gguf(path: Path, config: dict, n_layers: int, seed: int = 0) -> None:
    """Random StarCoder2 weights of ``config``'s sizes (N(0, 0.02) matrices and biases, LayerNorm
    scale 1 and shift 0) as a BF16 GGUF under the names the reference's loader reads
    (app/architectures/starcoder2.py:133-194)."""
    import torch
    from app.gguf.constants import GGMLQuantizationType
    from tools.make_tiny_gguf import GGUFBuilder

    h, heads, kv_heads = config["hidden_size"], config["num_attention_heads"], config["num_key_value_heads"]
    head_dim, inter, vocab = config["head_dim"], config["intermediate_size"], config["vocab_size"]
    builder = (GGUFBuilder()
               .set_str("general.architecture", "starcoder2")
               .set_u32("starcoder2.embedding_length", h)
               .set_u32("starcoder2.attention.head_count", heads)
               .set_u32("starcoder2.attention.head_count_kv", kv_heads)
               .set_u32("starcoder2.attention.key_length", head_dim)
               .set_u32("starcoder2.block_count", n_layers)
               .set_u32("starcoder2.feed_forward_length", inter)
               .set_f32("starcoder2.attention.layer_norm_epsilon", config["norm_epsilon"])
               .set_u32("starcoder2.vocab_size", vocab)
               .set_f32("starcoder2.rope.freq_base", config["rope_theta"]))
    generator = torch.Generator().manual_seed(seed)

    def add(name: str, shape: tuple[int, ...], kind: str) -> None:
        if kind == "ones":
            tensor = torch.ones(shape)
        elif kind == "zeros":
            tensor = torch.zeros(shape)
        else:
            tensor = torch.empty(shape).normal_(0.0, 0.02, generator=generator)
        raw = tensor.to(torch.bfloat16).view(torch.int16).numpy().tobytes()
        builder.add_tensor(name, list(reversed(shape)), GGMLQuantizationType.BF16, raw)

    add("token_embd.weight", (vocab, h), "normal")
    add("output_norm.weight", (h,), "ones")
    add("output_norm.bias", (h,), "zeros")
    if not config.get("tie_word_embeddings", True):
        add("output.weight", (vocab, h), "normal")
    q, kv = heads * head_dim, kv_heads * head_dim
    for layer in range(n_layers):
        p = f"blk.{layer}."
        for norm in ("attn_norm", "ffn_norm"):
            add(p + norm + ".weight", (h,), "ones")
            add(p + norm + ".bias", (h,), "zeros")
        for name, rows, cols in (("attn_q", q, h), ("attn_k", kv, h), ("attn_v", kv, h),
                                 ("attn_output", h, q), ("ffn_up", inter, h), ("ffn_down", h, inter)):
            add(p + name + ".weight", (rows, cols), "normal")
            add(p + name + ".bias", (rows,), "normal")
    builder.write(path)


def load_reference_model(config: dict, n_layers: int, device_spec: str):
    import torch
    from app.architectures.starcoder2 import Starcoder2Architecture
    from app.gguf.loader import GGUFModelLoader
    from app.runtime.compute_device import ComputeDevice

    device = ComputeDevice.resolve(device_spec)
    dtype = device.load_dtype() if device.is_gpu else torch.bfloat16
    with tempfile.TemporaryDirectory() as folder:
        path = Path(folder) / "starcoder2_random_bf16.gguf"
        write_random_gguf(path, config, n_layers)
        loader = GGUFModelLoader(path, dtype=dtype)
        model = Starcoder2Architecture.from_gguf(loader, dtype=dtype).eval()
        model.place_on(device.torch_device)
        with torch.no_grad():
            model.forward(torch.tensor([[1, 2, 3]], dtype=torch.long))     # copies the weights in
    return model, dtype


class Replies:
    """``batch`` requests driven the way the reference's worker drives them: each a
    ``stream_steps`` coroutine; their pending decode steps go to ``BatchDecoder.decode`` together."""

    def __init__(self, model, batch: int, prompt_len: int, vocab: int, num_predict: int, num_ctx: int,
                 seed: int) -> None:
        import torch
        from app.runtime.batch_decode import BatchDecoder, DecodeStep
        from app.runtime.chat_engine import ChatEngine
        from app.runtime.generation_request import GenerationRequest, SamplingConfig

        self._decode_step_type = DecodeStep
        self.decoder = BatchDecoder(model, max_batch=max(batch, 1))
        generator = torch.Generator().manual_seed(seed)
        sampling = SamplingConfig(temperature=0.0, top_p=1.0, top_k=0, repeat_penalty=1.0,
                                  num_ctx=num_ctx, num_predict=num_predict, seed=0)
        self.coroutines = []
        self.pending = []
        self.tokens_out = 0
        for _ in range(batch):
            ids = torch.randint(0, vocab, (1, prompt_len), generator=generator)
            steps = ChatEngine(model, set()).stream_steps(GenerationRequest(ids, sampling))
            self.coroutines.append(steps)
            self.pending.append(self._advance(steps, None, first=True))

    def _advance(self, steps, logits, first: bool = False):
        """Runs a coroutine until it asks for its next decode step (it yields checkpoints between
        prompt pieces and the sampled token before that)."""
        item = next(steps) if first else steps.send(logits)
        while not isinstance(item, self._decode_step_type):
            if isinstance(item, int):
                self.tokens_out += 1
            item = steps.send(None)
        return item

    def round(self, timer=None) -> None:
        """One decode step of every request: one ``BatchDecoder.decode`` call, then every coroutine
        takes its logits, samples on the host and hands in its next step."""
        if timer is not None:
            timer.begin()
        results = self.decoder.decode(self.pending)
        if timer is not None:
            timer.end()
        for index, (steps, result) in enumerate(zip(self.coroutines, results)):
            if isinstance(result, Exception):
                raise result
            self.pending[index] = self._advance(steps, result)

    def close(self) -> None:
        for steps in self.coroutines:
            steps.close()


class DeviceTimer:
    """CUDA events around each timed call, summed (wall clock on a CPU device)."""

    def __init__(self, cuda: bool) -> None:
        self.cuda = cuda
        self.pairs = []
        self.seconds = 0.0

    def begin(self) -> None:
        if self.cuda:
            import torch
            self._start = torch.cuda.Event(enable_timing=True)
            self._start.record()
        else:
            self._t0 = time.perf_counter()

    def end(self) -> None:
        if self.cuda:
            import torch
            stop = torch.cuda.Event(enable_timing=True)
            stop.record()
            self.pairs.append((self._start, stop))
        else:
            self.seconds += time.perf_counter() - self._t0

    def total_ms(self) -> float:
        if self.cuda:
            import torch
            torch.cuda.synchronize()
            return sum(a.elapsed_time(b) for a, b in self.pairs)
        return self.seconds * 1e3


def time_decode(model, batch: int, context: int, vocab: int, steps: int, warmup: int, num_ctx: int, cuda: bool):
    """(device ms per step, end-to-end tokens per second) of ``steps`` decode rounds at ``batch``."""
    import torch

    replies = Replies(model, batch, context, vocab, num_predict=warmup + steps + 4, num_ctx=num_ctx, seed=batch)
    try:
        for _ in range(warmup):
            replies.round()
        if cuda:
            torch.cuda.synchronize()
        timer = DeviceTimer(cuda)
        produced_before = replies.tokens_out
        t0 = time.perf_counter()
        for _ in range(steps):
            replies.round(timer)
        if cuda:
            torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        produced = replies.tokens_out - produced_before
        return timer.total_ms() / steps, produced / seconds
    finally:
        replies.close()


def time_prefill(model, tokens: int, vocab: int, num_ctx: int, cuda: bool, repeats: int = 3) -> float:
    """Milliseconds from a request of ``tokens`` prompt tokens to its first sampled token, through
    ``ChatEngine.stream_steps`` (its stock 256-token pieces); the median of ``repeats``."""
    import torch
    from app.runtime.chat_engine import ChatEngine
    from app.runtime.generation_request import GenerationRequest, SamplingConfig

    sampling = SamplingConfig(temperature=0.0, top_p=1.0, top_k=0, repeat_penalty=1.0, num_ctx=num_ctx,
                              num_predict=1, seed=0)
    times = []
    generator = torch.Generator().manual_seed(3)
    for _ in range(repeats + 1):
        ids = torch.randint(0, vocab, (1, tokens), generator=generator)
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps = ChatEngine(model, set()).stream_steps(GenerationRequest(ids, sampling))
        for item in steps:
            if isinstance(item, int):
                break
        steps.close()
        if cuda:
            torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1e3)
    return sorted(times[1:])[len(times[1:]) // 2]


def run(args, config: dict, context: int, prefill_tokens: int, num_ctx: int, clocks=None) -> dict:
    """The reference's numbers as one record in the shape of ``bench.py``'s line."""
    import_reference()
    import torch

    device_spec = os.environ.get("MATRICXON_DEVICE", "cuda")
    cuda = device_spec.startswith("cuda")
    n_layers = args.layers
    model, dtype = load_reference_model(config, n_layers, device_spec)
    vocab = config["vocab_size"]
    mark_a = clocks.mark() if clocks else 0
    ms_step, e2e = time_decode(model, args.batch, context, vocab, args.steps, args.warmup, num_ctx, cuda)
    mark_b = clocks.mark() if clocks else 0
    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            steps = max(4, args.steps // 8) if batch == 64 else max(8, args.steps // 2)
            ms, _ = time_decode(model, batch, context, vocab, steps, 3, num_ctx, cuda)
            points[f"decode_b{batch}"] = round(batch / (ms * 1e-3), 1)
    prefill = None
    if not args.skip_prefill:
        pf_ms = time_prefill(model, prefill_tokens, vocab, num_ctx, cuda)
        prefill = {"value": round(prefill_tokens / (pf_ms * 1e-3), 1), "tokens": prefill_tokens,
                   "ms": round(pf_ms, 3)}
    record = {
        "impl": "reference",
        "metric": "decode tok/s @ batch 8 (StarCoder2-3B bf16, one B200)",
        "value": round(args.batch / (ms_step * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": str(dtype).replace("torch.", "").replace("bfloat16", "bf16"),
        "data": "synthetic: seeded random weights N(0,0.02) as a BF16 GGUF, uniform random token ids",
        "config": {"model": "StarCoder2-3B layer sizes", "layers": n_layers, "layers_in_model": 30,
                   "hidden": config["hidden_size"], "heads": config["num_attention_heads"],
                   "kv_heads": config["num_key_value_heads"], "head_dim": config["head_dim"],
                   "intermediate": config["intermediate_size"], "vocab": vocab,
                   "tied": config.get("tie_word_embeddings", True), "global_batch": args.batch,
                   "seq_len": num_ctx, "decode_context": int(context + args.warmup + args.steps / 2),
                   "path": "ChatEngine.stream_steps + BatchDecoder.decode, stock code on " + device_spec,
                   "window": "none (the reference reads no sliding window)", "parallelism": "single GPU"},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "steps": args.steps,
                "h2d_bytes_per_step": args.batch * 16, "d2h_bytes_per_step": args.batch * vocab * 2},
        "gpu_launches": None,
        "points": points,
    }
    if prefill is not None:
        record["prefill"] = prefill
    if clocks is not None:
        record["clocks"] = clocks.summary(mark_a, mark_b)
    del model
    if cuda:
        torch.cuda.empty_cache()
    return record


if __name__ == "__main__":
    print(json.dumps({"note": "run through bench.py --impl reference"}))
