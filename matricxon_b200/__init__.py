"""A B200-native (sm_100a) inference engine for the StarCoder2 architecture.

Everything between a request's tokens and its next token on one GPU: typed
configuration and an architecture registry, safetensors weights, layers
assembled from parts, a paged key/value cache, one step function over mixed
batches, a scheduler, sampling, a Python entry point and a command line.

The public names mirror the reference engine's generation API
(app/runtime/chat_engine.py:17-210, app/runtime/generation_request.py:8-41):
``ChatEngine``, ``GenerationRequest``, ``SamplingConfig``, ``GenerationResult``.
"""

__version__ = "0.1.0"

_LAZY = {
    "ChatEngine": ("matricxon_b200.engine.chat_engine", "ChatEngine"),
    "GenerationRequest": ("matricxon_b200.engine.request", "GenerationRequest"),
    "GenerationResult": ("matricxon_b200.engine.request", "GenerationResult"),
    "SamplingConfig": ("matricxon_b200.sampling.config", "SamplingConfig"),
    "Starcoder2Config": ("matricxon_b200.config.starcoder2", "Starcoder2Config"),
    "load_config": ("matricxon_b200.config.registry", "load_config"),
    "write_random_model": ("matricxon_b200.weights.random_init", "write_random_model"),
}


def __getattr__(name):
    target = _LAZY.get(name)
    if target is None:
        raise AttributeError(f"module 'matricxon_b200' has no attribute {name!r}")
    import importlib

    return getattr(importlib.import_module(target[0]), target[1])
