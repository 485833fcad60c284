"""Device memory behind the cache manager: page storage per group, the state-slot slab."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from .manager import PagedNeed, StateLayout


class CacheStorage:
    """Keys and values of group g: ``k[g]``, ``v[g]`` of shape
    [layers of the group, pages, kv_heads, page_tokens, head_dim] (values: the need's ``value_dim`` as the
    last size, which may differ from the keys' or be 0) in the path's element type,
    so one (layer, page, head) tile is a contiguous [page_tokens, head_dim] box.
    Fixed-size state: ``state`` [slots, slot_elements] float32.

    Every group has some pages more than its pool gives out (``scratch_page_count`` of them, enough for 128
    positions, from ``scratch_pages[g]`` on), and the slab one slot more than the manager does
    (``scratch_slot``): rows that a step adds to reach a launch shape it has a captured graph for write there,
    and nothing ever reads them."""

    def __init__(self, groups: Sequence[Tuple[PagedNeed, int]], group_pages: Sequence[int], page_tokens: int,
                 state_layout: StateLayout, slots: int, dtype: torch.dtype, device: torch.device):
        self.page_tokens = page_tokens
        self.scratch_page_count = max(1, -(-128 // page_tokens))
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        for (need, layers), pages in zip(groups, group_pages):
            shape = (layers, pages + self.scratch_page_count, need.kv_heads, page_tokens, need.head_dim)
            value_shape = (layers, pages + self.scratch_page_count, need.kv_heads, page_tokens, need.value_dim)
            # zeros, not empty: a page that was never written must not hold NaN bit patterns,
            # because masked keys are still multiplied by a zero weight in some kernels
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros(value_shape, dtype=dtype, device=device))
        self.scratch_pages = [int(pages) for pages in group_pages]
        self.scratch_slot = int(slots)
        self.slot_elements = max(state_layout.slot_elements, 4)
        self.state = torch.zeros((slots + 1, self.slot_elements), dtype=torch.float32, device=device)

    def clear_slot(self, slot: int) -> None:
        self.state[slot].zero_()

    def bytes(self) -> int:
        total = self.state.numel() * 4
        for tensor in (*self.k, *self.v):
            total += tensor.numel() * tensor.element_size()
        return total
