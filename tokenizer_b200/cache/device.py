"""The device side of the cache: one pool of pages per group, one state arena
per call that declares state, and the bindings handed to the mixers."""
from __future__ import annotations

from typing import List

import torch

from ..parts.base import CacheBinding, Runtime
from .manager import CachePlan, RequestCache


class DeviceCache(CachePlan):
    """`CachePlan` plus the memory.  Pool of group g:
    [calls in the group, planes (keys, values; or one row for both), pages * page_size,
    kv_heads, head_dim] in the compute dtype; a token's keys of one call lie at row
    page * page_size + offset."""

    def __init__(self, needs, num_pages: int, page_size: int, max_requests: int,
                 runtime: Runtime, share_prefixes: bool = False):
        super().__init__(needs, num_pages, page_size, max_requests, share_prefixes)
        self.runtime = runtime
        self.pools: List[torch.Tensor] = []
        for layout in self.groups:
            self.pools.append(torch.zeros(
                (len(layout.calls), layout.planes, num_pages * page_size, layout.kv_heads, layout.head_dim),
                dtype=runtime.dtype, device=runtime.device))
        self.states = {}
        for call in self.state_calls:
            self.states[call] = torch.zeros(
                (max_requests,) + tuple(needs[call].state.shape), dtype=torch.float32,
                device=runtime.device)
        # what a layer's arrangement keeps beside its mixer's state: arenas of their own
        self.side_states = {}
        for call, need in enumerate(needs):
            side = getattr(need, "side_state", None) if need is not None else None
            if side is not None:
                self.side_states[call] = torch.zeros((max_requests,) + tuple(side.shape), dtype=torch.float32,
                                                     device=runtime.device)
        self._needs = needs

    def _arenas(self):
        return list(self.states.values()) + list(self.side_states.values())

    def on_open(self, cache: RequestCache) -> None:
        for arena in self._arenas():
            arena[cache.state_slot].zero_()

    def on_release(self, cache: RequestCache) -> None:
        if cache.length:            # a request that is recomputed from its first token starts from zero
            for arena in self._arenas():
                arena[cache.state_slot].zero_()

    def bindings(self, order) -> List[CacheBinding]:
        """One binding per call of the order."""
        out = []
        for at, call in enumerate(order):
            source = at if call.cache is None else call.cache
            group = self.group_of_call[source]
            binding = CacheBinding(writes=call.cache is None)
            if group is not None:
                layer = self.groups[group].calls.index(source)
                binding.group = group
                binding.k_pool = self.pools[group][layer, 0]
                binding.v_pool = self.pools[group][layer, 1] if self.groups[group].planes > 1 else None
            binding.state = self.states.get(source)
            binding.side_state = self.side_states.get(source)
            out.append(binding)
        return out

    def bytes_per_token(self) -> int:
        size = torch.empty((), dtype=self.runtime.dtype).element_size()
        return sum(len(g.calls) * g.planes * g.kv_heads * g.head_dim * size for g in self.groups)
