"""Where the one-kernel decode step (csrc/decode_fused.cu) spends its time.

    MATRICXON_NVCC_EXTRA=-DDF_PROFILE MATRICXON_FUSED_DECODE=1 \
        python -m matricxon_b200.ops.fused_profile [layers] [batch]

Builds the library with the kernel's cycle counters compiled in, runs decode steps of a
StarCoder2-3B-sized model with random weights (``layers`` layers, ``batch`` requests at about
3,000 cached tokens) and prints, per block and step, the microseconds thread 0 of the consumer
warps spent in each part of the kernel and the producer warp spent waiting for a free slot.
"""
import ctypes
import sys

import numpy as np
import torch

NAMES = ["combine_stats", "chunk_loops", "grid_barriers", "stage_activations", "unit_epilogues",
         "attention", "merge_splits", "producer_wait_free_slot", "consumer_wait_chunk", "kernel_total",
         "producer_total", "producer_wait_new_kv"]
SIZES = {"model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"], "hidden_size": 3072,
         "num_attention_heads": 24, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 12288,
         "vocab_size": 49152, "rope_theta": 999999.4420358813, "sliding_window": 4096,
         "max_position_embeddings": 16384, "norm_epsilon": 1e-5, "use_bias": True,
         "tie_word_embeddings": True, "hidden_act": "gelu_pytorch_tanh"}


def main() -> None:
    from matricxon_b200.config.registry import config_from_dict
    from matricxon_b200.engine.core import EngineCore, build_model
    from matricxon_b200.engine.step import StepEntry
    from matricxon_b200.ops.library import KernelLibraryError, library
    from matricxon_b200.weights.random_init import RandomInit, RandomSource, weight_specs_for

    layers = int(sys.argv[1]) if len(sys.argv) > 1 else 4
    batch = int(sys.argv[2]) if len(sys.argv) > 2 else 8
    lib = library()
    if not hasattr(lib, "mx_decode_fused_profile"):
        raise KernelLibraryError("build with MATRICXON_NVCC_EXTRA=-DDF_PROFILE to get the counters")
    lib.mx_decode_fused_profile.argtypes = [ctypes.c_void_p, ctypes.c_int]
    config = config_from_dict(dict(SIZES, num_hidden_layers=layers))
    source = RandomSource(weight_specs_for(config), seed=0, init=RandomInit(0.02, 0.02), device="cuda:0",
                          store_dtype=torch.bfloat16)
    model = build_model(config, source, "bfloat16", "cuda:0", 16)
    core = EngineCore(model, max_cache_tokens=batch * 4096, max_requests=batch, max_model_len=4096)
    if core.runner.fused is None:
        raise KernelLibraryError("the fused decode step is off: set MATRICXON_FUSED_DECODE=1")
    generator = torch.Generator().manual_seed(1)
    ids = [f"r{i}" for i in range(batch)]
    for rid in ids:
        core.cache.add_request(rid)
        for start in range(0, 3000, 1000):
            core.runner.run([StepEntry(rid, torch.randint(0, 49152, (1000,), generator=generator).tolist(), [])])

    def decode(steps: int) -> float:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for _ in range(steps):
            tokens = torch.randint(0, 49152, (batch,), generator=generator).tolist()
            core.runner.run([StepEntry(rid, [tok], [0]) for rid, tok in zip(ids, tokens)])
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) * 1e3 / steps

    decode(6)
    lib.mx_decode_fused_profile(None, 1)
    steps = 16
    per_step = decode(steps)
    core.runner.check_status()
    out = np.zeros((256, 16), dtype=np.uint64)
    lib.mx_decode_fused_profile(out.ctypes.data, 0)
    props = torch.cuda.get_device_properties(0)
    try:
        ghz = torch.cuda.clock_rate() / 1e3          # the SM clock right after the timed steps
    except Exception:
        ghz = 1.965
    per = out[:props.multi_processor_count].astype(np.float64) / steps / ghz / 1e3
    print(f"{layers} layers + head, batch {batch}: {per_step:.1f} us per step (counters on; SM clock taken as {ghz:.3f} GHz)")
    print(f"{'part':28s} {'mean us':>9s} {'min':>9s} {'max':>9s} {'per layer':>10s}")
    for index, name in enumerate(NAMES):
        column = per[:, index]
        print(f"{name:28s} {column.mean():9.1f} {column.min():9.1f} {column.max():9.1f} {column.mean() / layers:10.2f}")


if __name__ == "__main__":
    main()
