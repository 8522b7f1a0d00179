"""Seeded random weights for any registered configuration, and a writer of model folders.

The reference only draws random weights in its tests: ``N(0, 0.02)`` matrices and biases,
norm scales ``1 + N(0, 0.05)``, from ``np.random.RandomState(seed)``
(tests/tiny_gguf_starcoder2.py:32-45). Here each tensor is drawn from its own generator
seeded by (seed, position of the tensor in the model's weight list), so one tensor can be
reproduced without drawing the others, on the CPU or directly on a GPU.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from matricxon_b200.config.registry import entry_for_config
from matricxon_b200.weights.loader import WeightSpec
from matricxon_b200.weights.safetensors_io import write_safetensors


@dataclass(frozen=True)
class RandomInit:
    weight_std: float = 0.02
    bias_std: float = 0.02
    norm_weight_std: float = 0.0      # scale is 1 + N(0, std)
    norm_bias_std: float = 0.0


def weight_specs_for(config) -> list[WeightSpec]:
    from matricxon_b200.models.decoder import model_weight_specs

    entry_for_config(config)   # fails for an unregistered configuration
    return model_weight_specs(config.model_spec())


class RandomSource:
    """A TensorSource that draws each tensor when it is read."""

    def __init__(self, specs: list[WeightSpec], seed: int, init: RandomInit = RandomInit(),
                 device: str | torch.device = "cpu", store_dtype: torch.dtype = torch.float32) -> None:
        self.specs = {spec.name: (index, spec) for index, spec in enumerate(specs)}
        self.seed = seed
        self.init = init
        self.device = torch.device(device)
        self.store_dtype = store_dtype

    def names(self) -> list[str]:
        return list(self.specs)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.specs[name][1].shape)

    def dtype(self, name: str) -> torch.dtype:
        return torch.int32 if self.specs[name][1].role == "int_table" else self.store_dtype

    def read(self, name: str) -> torch.Tensor:
        index, spec = self.specs[name]
        generator = torch.Generator(device=self.device)
        generator.manual_seed((self.seed * 1_000_003 + index) & 0x7FFFFFFFFFFFFFFF)
        if spec.role == "int_table":
            return torch.zeros(spec.shape, dtype=torch.int32, device=self.device)
        std, mean = {"weight": (self.init.weight_std, 0.0), "bias": (self.init.bias_std, 0.0),
                     "norm_weight": (self.init.norm_weight_std, 1.0),
                     "norm_bias": (self.init.norm_bias_std, 0.0)}[spec.init]
        if std == 0.0:
            values = torch.full(spec.shape, mean, dtype=torch.float32, device=self.device)
        else:
            values = torch.randn(spec.shape, generator=generator, dtype=torch.float32,
                                 device=self.device) * std + mean
        return values.to(self.store_dtype)


def random_tensors(config, seed: int, init: RandomInit = RandomInit(),
                   store_dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    source = RandomSource(weight_specs_for(config), seed, init, "cpu", store_dtype)
    return {name: source.read(name) for name in source.names()}


def write_random_model(folder: str | Path, config, seed: int, init: RandomInit = RandomInit(),
                       store_dtype: torch.dtype | str = torch.float32) -> Path:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` with seeded weights."""
    if isinstance(store_dtype, str):
        store_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[store_dtype]
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = "bfloat16" if store_dtype == torch.bfloat16 else "float32"
    with open(folder / "config.json", "w", encoding="utf-8") as handle:
        json.dump(raw, handle, indent=2, sort_keys=True)
        handle.write("\n")
    source = RandomSource(weight_specs_for(config), seed, init, "cpu", store_dtype)
    write_safetensors(folder / "model.safetensors",
                      ((name, source.read(name)) for name in source.names()),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
