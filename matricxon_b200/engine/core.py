"""Assembly of a runnable engine core: model + cache manager + cache storage + step runner.

The reference's ModelManager builds a handle of architecture, worker and prompt cache
from a file (app/models/manager.py:306-435) and picks bf16 on a GPU
(app/runtime/compute_device.py:74-79). Here a model folder (config.json +
model.safetensors), or tensors already in memory, become a ``DecoderModel`` on one
CUDA device with a paged cache sized in tokens.
"""

from __future__ import annotations

from pathlib import Path

import torch

from matricxon_b200.cache.manager import CacheManager, GroupRule
from matricxon_b200.cache.storage import CacheStorage, bytes_per_token
from matricxon_b200.config.registry import entry_for_config, load_config
from matricxon_b200.engine.step import StepRunner
from matricxon_b200.ops.library import KernelLibraryError, library
from matricxon_b200.parts.base import Runtime
from matricxon_b200.weights.loader import DictSource, make_fetcher
from matricxon_b200.weights.safetensors_io import ModelFiles

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name: str | torch.dtype) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not {name!r}") from None


def _require_gpu(device: torch.device) -> None:
    if device.type != "cuda":
        raise KernelLibraryError(f"the engine runs on a CUDA device only, not {device}")
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device is available; the engine has no CPU path")
    library()   # build or load the kernels now, loudly


def build_model(config, source, dtype, device="cuda:0", page_size: int = 16,
                gemm_backend: str = "auto"):
    """The registered model of ``config`` with weights from ``source`` (a TensorSource)."""
    device = torch.device(device)
    _require_gpu(device)
    runtime = Runtime(device=device, dtype=parse_dtype(dtype), page_size=page_size,
                      gemm_backend=gemm_backend)
    model = entry_for_config(config).build_model(config, runtime)
    fetch = make_fetcher(model.weight_specs(), source, runtime.dtype, device)
    model.load(fetch)
    return model


def load_model(model_dir: str | Path, dtype="bfloat16", device="cuda:0", page_size: int = 16,
               gemm_backend: str = "auto"):
    """(config, model) from a folder with config.json and model.safetensors."""
    config = load_config(model_dir)
    model = build_model(config, ModelFiles(model_dir), dtype, device, page_size, gemm_backend)
    return config, model


def model_from_tensors(config, tensors: dict[str, torch.Tensor], dtype="bfloat16",
                       device="cuda:0", page_size: int = 16, gemm_backend: str = "auto"):
    return build_model(config, DictSource(tensors), dtype, device, page_size, gemm_backend)


class EngineCore:
    """A model with its cache: what the scheduler, the entry point and trace replay drive."""

    def __init__(self, model, max_cache_tokens: int, max_requests: int = 64,
                 max_step_tokens: int = 8192, poison_cache: bool = False,
                 max_model_len: int | None = None, use_graphs: bool = True) -> None:
        runtime = model.runtime
        plan = model.cache_plan
        page_size = runtime.page_size
        pages = max(1, (max_cache_tokens + page_size - 1) // page_size)
        pages_per_group = [pages for _ in plan.groups]
        self.model = model
        self.page_size = page_size
        self.cache = CacheManager([GroupRule(window=g.request.window) for g in plan.groups],
                                  pages_per_group, page_size, max_requests)
        self.storage = CacheStorage(plan, pages_per_group, page_size, runtime.dtype,
                                    runtime.device, max_requests, poison=poison_cache)
        self.runner = StepRunner(model, self.cache, self.storage, max_step_tokens=max_step_tokens,
                                 max_step_seqs=max(max_requests, 1), max_model_len=max_model_len,
                                 use_graphs=use_graphs)
        self.bytes_per_token = bytes_per_token(plan, runtime.dtype)
