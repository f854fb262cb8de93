"""Device memory behind the cache manager's page ids and state slots.

The reference keeps one pool ``[L, 2, num_blocks, block_size, n_kv, d]`` (csrc/executor/kv_cache.cpp:9-25).
Here every cache group has a pool ``[runs, pages, planes, n_kv, page_size, d]`` (planes: keys and values, or the one
row of a mixer that caches a latent): the keys (or values) of one page and one kv head are ``page_size * d``
contiguous elements, which is the tile an attention kernel loads.  Per-request state of fixed size lives in ``[slots, *shape]`` tensors, one per run that asks for it.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..parts.spec import StateNeed
from .manager import CacheGroupSpec

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


def page_bytes(group: CacheGroupSpec, page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page id stands for: keys and values of every run of the group."""
    width = torch.empty((), dtype=dtype).element_size()
    return len(group.runs) * group.planes * group.num_kv_heads * page_size * group.head_dim * width


class CacheStorage:
    def __init__(self, groups: Sequence[CacheGroupSpec], page_size: int, num_pages: Sequence[int],
                 state_needs: Dict[int, StateNeed], max_requests: int, dtype: torch.dtype, device) -> None:
        self.page_size = page_size
        self.dtype = dtype
        self.pools: List[torch.Tensor] = []
        self.run_cache: Dict[int, torch.Tensor] = {}
        self.run_group: Dict[int, int] = {}
        for g, (spec, pages) in enumerate(zip(groups, num_pages)):
            pool = torch.zeros((len(spec.runs), pages, spec.planes, spec.num_kv_heads, page_size, spec.head_dim),
                               dtype=dtype, device=device)
            self.pools.append(pool)
            for i, run in enumerate(spec.runs):
                self.run_cache[run] = pool[i]
                self.run_group[run] = g
        self.state: Dict[int, object] = {}          # run -> tensor, or name -> tensor for a mixer with several

        def make(need: StateNeed) -> torch.Tensor:
            if need.dtype not in _STATE_DTYPES:
                raise ValueError(f"state dtype {need.dtype!r} is not one of {sorted(_STATE_DTYPES)}")
            return torch.zeros((max_requests, *need.shape), dtype=_STATE_DTYPES[need.dtype], device=device)

        for run, need in state_needs.items():
            if isinstance(need, (tuple, list)):
                if len({n.name for n in need}) != len(need) or not all(n.name for n in need):
                    raise ValueError(f"run {run}: several state tensors need a name each")
                self.state[run] = {n.name: make(n) for n in need}
            else:
                self.state[run] = make(need)

    def state_tensors(self) -> List[torch.Tensor]:
        out: List[torch.Tensor] = []
        for entry in self.state.values():
            out.extend(entry.values() if isinstance(entry, dict) else [entry])
        return out

    def zero_slots(self, slots: Sequence[int]) -> None:
        """A request that has just been admitted starts from zero state."""
        tensors = self.state_tensors()
        if not slots or not tensors:
            return
        idx = torch.tensor(list(slots), dtype=torch.long, device=tensors[0].device)
        for t in tensors:
            t.index_fill_(0, idx, 0)
