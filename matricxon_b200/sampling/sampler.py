"""Per-request sampling state on the host, one kernel launch per step on the device.

The reference gives every request its own ``torch.Generator`` and draws one uniform per
token (app/runtime/sampler.py:87-98). Here the uniform of a request's n-th token is a
pure function of (seed, n): a request draws the same numbers whatever else is in the
batch, and a request that was preempted and recomputed continues its stream unchanged.
"""

from __future__ import annotations

import os

import numpy as np
import torch

from matricxon_b200.ops import kernels
from matricxon_b200.ops.library import check, library, register_signature
from matricxon_b200.sampling.config import SamplingConfig

from ctypes import c_int, c_longlong, c_void_p

register_signature("mx_sample_scratch_bytes", [c_int, c_int], c_longlong)
register_signature("mx_sample", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p], c_int)

_MASK = (1 << 64) - 1


def uniform_for(seed: int, counter: int) -> float:
    """A uniform in [0, 1) with 24 bits from (seed, counter): splitmix64 of their mix."""
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


class RequestSampler:
    """What one request needs to pick its tokens: options, stream position, generated ids."""

    def __init__(self, config: SamplingConfig) -> None:
        self.config = config
        self.seed = config.seed if config.seed is not None else int.from_bytes(os.urandom(8), "little")
        self.generated: list[int] = []
        self._distinct: set[int] = set()
        self._distinct_list: list[int] = []

    def next_uniform(self) -> float:
        return uniform_for(self.seed, len(self.generated))

    def accept(self, token: int) -> None:
        self.generated.append(token)
        if token not in self._distinct:
            self._distinct.add(token)
            self._distinct_list.append(token)

    def penalty_ids(self) -> list[int]:
        if self.config.repeat_penalty == 1.0:
            return []
        return self._distinct_list


class BatchSampler:
    """Chooses one token per logits row on the device and brings the ids to the host."""

    def __init__(self, device: torch.device, vocab_size: int) -> None:
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self._work: torch.Tensor | None = None
        self._params_host: torch.Tensor | None = None
        self._params_dev: torch.Tensor | None = None
        self._params_done: torch.cuda.Event | None = None
        self.last_upload_bytes = 0

    def sample(self, logits: torch.Tensor, samplers: list[RequestSampler]) -> list[int]:
        """``logits`` float32 [rows, vocab] on the device; returns the chosen ids (a device
        synchronisation) without recording them: callers ``accept`` what they keep."""
        n = len(samplers)
        if logits.shape[0] != n or logits.shape[1] != self.vocab_size:
            raise ValueError(f"logits {tuple(logits.shape)} for {n} requests, vocab {self.vocab_size}")
        if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
            raise ValueError("logits must be float32 on the CUDA device with unit column stride")
        # one int32 buffer: temperature, top_p, repeat_penalty, uniform (float bits), then top_k,
        # penalty offsets, penalty ids; one pinned copy to the device
        offsets = [0]
        ids: list[int] = []
        for s in samplers:
            ids.extend(s.penalty_ids())
            offsets.append(len(ids))
        total = 4 * n + n + (n + 1) + len(ids)
        packed = np.empty(total, dtype=np.int32)
        as_float = packed[:4 * n].view(np.float32)
        as_float[0:n] = [s.config.temperature for s in samplers]
        as_float[n:2 * n] = [s.config.top_p for s in samplers]
        as_float[2 * n:3 * n] = [s.config.repeat_penalty for s in samplers]
        as_float[3 * n:4 * n] = [s.next_uniform() for s in samplers]
        packed[4 * n:5 * n] = [s.config.top_k for s in samplers]
        packed[5 * n:6 * n + 1] = offsets
        if ids:
            packed[6 * n + 1:] = ids
        if self._params_host is None or self._params_host.numel() < total:
            size = max(total, 4096)
            self._params_host = torch.empty(size, dtype=torch.int32, pin_memory=True)
            self._params_dev = torch.empty(size, dtype=torch.int32, device=self.device)
            self._params_done = torch.cuda.Event()
        self._params_done.synchronize()
        self._params_host[:total].copy_(torch.from_numpy(packed))
        self._params_dev[:total].copy_(self._params_host[:total], non_blocking=True)
        self._params_done.record()
        self.last_upload_bytes = total * 4
        if self._work is None or self._work.numel() < n * self.vocab_size:
            self._work = torch.empty(max(n, 8) * self.vocab_size, dtype=torch.float32, device=self.device)
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        base = self._params_dev.data_ptr()
        check(library().mx_sample(
            logits.data_ptr(), logits.stride(0), n, self.vocab_size,
            base, base + 4 * (4 * n), base + 4 * n, base + 4 * (2 * n), base + 4 * (3 * n),
            base + 4 * (5 * n), base + 4 * (6 * n + 1), self._work.data_ptr(), out.data_ptr(),
            torch.cuda.current_stream().cuda_stream), "sample")
        kernels._launched()
        return out.cpu().tolist()
