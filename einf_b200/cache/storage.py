"""Device storage behind the cache plan of a model.

Every schedule entry that owns a paged cache gets one tensor
``[2, pages, kv_heads, page_size, head_size]`` (keys, values): a page of one
key/value head is ``page_size * head_size`` contiguous elements, which is the
tile the attention kernels stream.  Pages of one group share their numbering
across the layers of the group, so one block table per request serves them all
(as the single geometry of the reference does,
``src/einf/cache/storage.py:52-85``).  Entries with a state need get
``[slots, *shape]``, zeroed when a request starts.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..parts.base import CacheView, PagedKVNeed, StateNeed
from ..parts.model import CachePlan


class CacheStorage:
    def __init__(
        self,
        plan: CachePlan,
        pages_per_group: Sequence[int],
        page_size: int,
        num_state_slots: int,
        dtype: torch.dtype,
        device: torch.device | str,
    ) -> None:
        if len(pages_per_group) != len(plan.group_windows):
            raise ValueError("one page count per cache group is needed")
        self.plan = plan
        self.page_size = page_size
        self.pages_per_group = tuple(pages_per_group)
        self.num_state_slots = num_state_slots
        self._owned: dict[int, torch.Tensor] = {}
        self.views: list[CacheView] = []
        for index, entry in enumerate(plan.entries):
            need = entry.need
            if entry.owner == index and isinstance(need, PagedKVNeed):
                self._owned[index] = torch.zeros(
                    (2, self.pages_per_group[entry.group], need.num_kv_heads, page_size, need.head_size),
                    dtype=dtype,
                    device=device,
                )
            elif entry.owner == index and isinstance(need, StateNeed):
                if num_state_slots <= 0:
                    raise ValueError("the model has per-request state but the engine has no state slots")
                self._owned[index] = torch.zeros((num_state_slots, *need.shape), dtype=need.dtype, device=device)
        for index, entry in enumerate(plan.entries):
            need = entry.need
            if isinstance(need, PagedKVNeed):
                kv = self._owned[entry.owner]
                self.views.append(
                    CacheView(group=entry.group, k=kv[0], v=kv[1], writes=entry.owner == index, page_size=page_size)
                )
            elif isinstance(need, StateNeed):
                self.views.append(CacheView(state=self._owned[entry.owner], writes=entry.owner == index))
            else:
                self.views.append(CacheView(writes=False))

    @property
    def state_tensors(self) -> list[torch.Tensor]:
        return [t for i, t in self._owned.items() if isinstance(self.plan.entries[i].need, StateNeed)]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._owned.values())
