"""Device tensors behind the cache manager's page numbers and state slots.

One allocation per group: [entries, pages, planes, kv heads, page_size * head_dim] in the
runtime dtype (kept 6-D as [..., page_size, head_dim] for its element count), ``planes`` being
what the group's mixers asked for (two for attention: keys and values). What lies inside a
tile is the mixer's convention, not this file's. The attention part keeps one page's keys for
one KV head as a contiguous ``[slot][dim]`` tile and its values transposed as ``[dim][slot]``,
which lets a tensor-core kernel read the keys of one value dimension with one 16-byte load;
``keys_view`` / ``values_view`` give those two layouts names. Fixed-size state: one tensor [slots, *shape] per
schedule entry that asks for it (the reference allocates conv/ssm state per
recurrent layer the same way, app/runtime/mamba_cache.py:63-70).
"""

from __future__ import annotations

import torch

from matricxon_b200.models.decoder import CachePlan


class CacheStorage:
    def __init__(self, plan: CachePlan, pages_per_group: list[int], page_size: int,
                 dtype: torch.dtype, device: torch.device, num_state_slots: int,
                 poison: bool = False) -> None:
        self.plan = plan
        self.page_size = page_size
        self.groups: list[torch.Tensor] = []
        for group, pages in zip(plan.groups, pages_per_group):
            shape = (len(group.entries), pages, group.request.planes, group.request.num_kv_heads,
                     page_size, group.request.head_dim)
            tensor = torch.empty(shape, dtype=dtype, device=device)
            # NaN everywhere when asked: a read of a slot that was never written then shows
            tensor.fill_(float("nan")) if poison else tensor.zero_()
            self.groups.append(tensor)
        self.states: list[torch.Tensor | None] = []
        for request in plan.state_of_entry:
            if request is None:
                self.states.append(None)
            else:
                self.states.append(torch.zeros((num_state_slots, *request.shape),
                                               dtype=request.dtype, device=device))

    def zero_state(self, slot: int) -> None:
        """A slot handed to a new request starts from zero."""
        for state in self.states:
            if state is not None:
                state[slot].zero_()

    def bytes(self) -> int:
        total = sum(t.numel() * t.element_size() for t in self.groups)
        total += sum(t.numel() * t.element_size() for t in self.states if t is not None)
        return total


def keys_view(entry_cache: torch.Tensor) -> torch.Tensor:
    """[pages, kv heads, page_size, head_dim] view of the keys of one schedule entry's cache."""
    return entry_cache[:, 0]


def values_view(entry_cache: torch.Tensor) -> torch.Tensor:
    """[pages, kv heads, head_dim, page_size] view of the (transposed) values."""
    pages, _, heads, page_size, dim = entry_cache.shape
    return entry_cache[:, 1].reshape(pages, heads, page_size * dim).view(pages, heads, dim, page_size)


def bytes_per_token(plan: CachePlan, dtype: torch.dtype) -> int:
    width = torch.empty((), dtype=dtype).element_size()
    return sum(len(g.entries) * g.request.planes * g.request.num_kv_heads * g.request.head_dim * width
               for g in plan.groups)
