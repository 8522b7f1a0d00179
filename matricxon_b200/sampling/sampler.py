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
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
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

    def next_uniform(self, ahead: int = 0) -> float:
        """The uniform of the next token, or of the one ``ahead`` tokens after it."""
        return uniform_for(self.seed, len(self.generated) + ahead)

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
        self._results: list = [None, None]
        self._device_ids: list = [None, None]
        self._turn = 0

    def sample(self, logits: torch.Tensor, samplers: list[RequestSampler]) -> list[int]:
        """``logits`` float32 [rows, vocab] on the device; returns the chosen ids (a device
        synchronisation) without recording them: callers ``accept`` what they keep."""
        return self.read(self.launch(logits, samplers))

    def read(self, handle) -> list[int]:
        """Waits for the ids of ``launch`` (only for the work queued up to that launch)."""
        host, done, n = handle
        done.synchronize()
        return host[:n].tolist()

    def launch(self, logits: torch.Tensor, samplers: list[RequestSampler],
               pending: torch.Tensor | None = None):
        """Queues the sampling kernel and the copy of its ids to pinned host memory; returns a
        handle for ``read``. The ids also stay on the device in ``handle_ids(handle)``.

        ``pending`` (int32 [rows], on the device) holds, per row, a token that the request has
        generated but the host has not seen yet (the step before is still in flight): the
        kernel counts it among the request's generated ids for the repeat penalty, and the
        uniforms are the ones that follow it."""
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
        ahead = 0 if pending is None else 1
        as_float[3 * n:4 * n] = [s.next_uniform(ahead) for s in samplers]
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
        if pending is not None and (pending.dtype != torch.int32 or not pending.is_cuda or pending.numel() < n):
            raise ValueError("pending ids must be int32 on the device, one per row")
        check(library().mx_sample(
            logits.data_ptr(), logits.stride(0), n, self.vocab_size,
            base, base + 4 * (4 * n), base + 4 * n, base + 4 * (2 * n), base + 4 * (3 * n),
            base + 4 * (5 * n), base + 4 * (6 * n + 1),
            pending.data_ptr() if pending is not None else None, self._work.data_ptr(), out.data_ptr(),
            kernels._stream()), "sample")
        kernels._launched()
        # two result buffers in turn: a step may be launched before the ids of the one before are read
        self._turn ^= 1
        slot = self._results[self._turn]
        if slot is None or slot[0].numel() < n:
            slot = (torch.empty(max(n, 64), dtype=torch.int32, pin_memory=True), torch.cuda.Event())
            self._results[self._turn] = slot
        host, done = slot
        host[:n].copy_(out, non_blocking=True)
        done.record()
        self._device_ids[self._turn] = out
        return host, done, n

    def device_ids(self) -> torch.Tensor:
        """The ids of the latest ``launch`` on the device (int32 [rows])."""
        return self._device_ids[self._turn]
