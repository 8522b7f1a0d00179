"""What each kernel of a decode step costs in place: the captured step with that kernel launched twice.

    python -m matricxon_b200.ops.insitu_bench [batch]        # from the repository root (uses bench.py)

Builds the benchmark's model (StarCoder2-3B layer sizes, 30 layers, random weights), fills ``batch``
(default 8) requests to 3,000 cached tokens, times the captured decode step, then re-captures it with
one kernel at a time launched twice per call and prints the difference per layer. The second launch
repeats the first one's work on the same data (the residual products add twice: only the time is
meaningful); small matrices may be served from L2 the second time, so read the figures as lower bounds.
"""
import sys

import bench
from matricxon_b200.ops import kernels


def main() -> None:
    batch = int(sys.argv[1]) if len(sys.argv) > 1 else 8
    config, _model, engine = bench.build_engine(bench.STARCODER2_3B, 30, 64, 64 * bench.CONTEXT, 8192)
    ids = bench.fill_cache(engine, batch, 3000, config.vocab_size)
    runner = engine.core.runner
    layers = config.num_hidden_layers

    def timed(label: str) -> float:
        runner._graphs.clear()                      # the next step captures anew, with the patched launcher
        runner._graph_pool = None                   # (the graphs' memory pool goes with the last of them)
        ms = bench.time_decode(engine, ids, config.vocab_size, 24, 4)
        print(f"{label:26s} {ms * 1000:9.1f} us a step", flush=True)
        return ms

    def twice(name, condition=None):
        original = getattr(kernels, name)

        def doubled(*args, **kwargs):
            result = original(*args, **kwargs)
            if condition is None or condition(*args, **kwargs):
                original(*args, **kwargs)
            return result
        setattr(kernels, name, doubled)
        return lambda: setattr(kernels, name, original)

    def weight_is(n, k_dim):
        return lambda a, w, *rest, **kw: tuple(w.shape) == (n, k_dim)

    h, i = config.hidden_size, config.intermediate_size
    base = timed("plain step")
    cases = [("LayerNorm (both)", "layernorm", None), ("QKV + rotation", "gemm_skinny_rope", None),
             ("attention + merge", "paged_attention_mma", None), ("O", "gemm_skinny", weight_is(h, h)),
             ("library product (17-128 rows)", "epilogue", None),
             ("c_fc", "gemm_skinny", weight_is(i, h)), ("c_proj", "gemm_skinny", weight_is(h, i)),
             ("head (once a step)", "gemm_skinny", lambda a, w, *r, **kw: w.shape[0] == config.vocab_size)]
    for label, name, condition in cases:
        restore = twice(name, condition)
        try:
            ms = timed(label + " twice")
        finally:
            restore()
        print(f"    -> {(ms - base) * 1000:8.1f} us a step, {(ms - base) * 1000 / layers:6.2f} us a layer")
    timed("plain step again")


if __name__ == "__main__":
    main()
