"""The cache's device tensors and the views that mixers get of them.

For every layer run whose mixer keeps keys and values: one tensor
[num_pages, 2 (K, V), kv_heads, page_size, head_dim] in the engine's dtype, indexed by the
page ids of the run's group.  Inside a page each KV head's tokens are contiguous, so a
decode kernel streams page_size * head_dim elements per head in one piece.  (The reference
keeps [2, layers, pages, page_size, kv_heads, head_dim], nanovllm/engine/model_runner.py:870-881.)
For every run with fixed-size state: one zeroed tensor [num_slots, *shape].
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import CacheView, CompositeNeed, FixedStateNeed, PagedKVNeed, SharedPagesNeed, need_leaves
from .manager import GroupSpec


leaves = need_leaves


@dataclass
class CacheLayout:
    """Which group each run belongs to (None: the run keeps no pages).  A run whose mixer keeps several things
    (:class:`CompositeNeed`) has one entry per thing in ``leaf_group``; ``run_group`` names its first paged one."""
    groups: list[GroupSpec]
    run_group: list[int | None]
    needs: list
    leaf_group: list[list[int | None]] | None = None

    @classmethod
    def from_needs(cls, needs: list) -> "CacheLayout":
        groups: list[GroupSpec] = []
        run_group: list[int | None] = []
        leaf_group: list[list[int | None]] = []
        for need in needs:
            mine: list[int | None] = []
            for leaf in leaves(need):
                if isinstance(leaf, PagedKVNeed):
                    g = GroupSpec(leaf.window, leaf.chunk, leaf.keep_first if leaf.window is not None else 0)
                    if g not in groups:
                        groups.append(g)
                    mine.append(groups.index(g))
                else:
                    mine.append(None)
            leaf_group.append(mine)
            run_group.append(next((g for g in mine if g is not None), None))
        return cls(groups, run_group, list(needs), leaf_group)

    @property
    def needs_state_slots(self) -> bool:
        return any(isinstance(leaf, FixedStateNeed) for n in self.needs for leaf in leaves(n))

    def page_bytes(self, page_size: int, dtype: torch.dtype) -> list[int]:
        """Bytes that one page id of each group stands for (summed over the group's runs)."""
        item = torch.empty((), dtype=dtype).element_size()
        out = [0] * len(self.groups)
        for need, groups in zip(self.needs, self.leaf_group):
            for leaf, g in zip(leaves(need), groups):
                if g is not None:
                    out[g] += leaf.planes * leaf.num_kv_heads * page_size * leaf.row_dim * item
        return out

    def state_bytes_per_slot(self, dtype: torch.dtype) -> int:
        total = 0
        for need in self.needs:
            for leaf in leaves(need):
                if isinstance(leaf, FixedStateNeed):
                    n = 1
                    for s in leaf.shape:
                        n *= s
                    total += n * (4 if leaf.dtype == "float32" else torch.empty((), dtype=dtype).element_size())
        return total


class CacheStorage:
    def __init__(self, layout: CacheLayout, order, page_size: int, num_pages: list[int], num_state_slots: int,
                 dtype: torch.dtype, device, poison: bool = False):
        """``poison``: the pools start as NaN instead of zeros, so that a kernel that reads a slot which no step
        has written (beyond a request's tokens, or a page of another request) cannot go unnoticed."""
        self.layout = layout
        self.order = list(order)
        self.page_size = page_size
        self.num_pages = list(num_pages)
        fill = float("nan") if poison else 0.0
        # per run, per leaf of its need: (pages, state); ``pages`` / ``states`` keep the first of each kind per run
        self.leaf_tensors: list[list[tuple]] = []
        self.pages: list[torch.Tensor | None] = []
        self.states: list[torch.Tensor | None] = []
        for need, groups in zip(layout.needs, layout.leaf_group):
            mine = []
            for leaf, g in zip(leaves(need), groups):
                if isinstance(leaf, PagedKVNeed):
                    mine.append((torch.full((num_pages[g], leaf.planes, leaf.num_kv_heads, page_size, leaf.row_dim), fill,
                                            dtype=dtype, device=device), None))
                elif isinstance(leaf, SharedPagesNeed):
                    mine.append((None, None))
                else:
                    sdt = torch.float32 if leaf.dtype == "float32" else dtype
                    mine.append((None, torch.full((max(num_state_slots, 1), *leaf.shape), fill, dtype=sdt,
                                                  device=device)))
            self.leaf_tensors.append(mine)
            self.pages.append(next((p for p, _ in mine if p is not None), None))
            self.states.append(next((s for _, s in mine if s is not None), None))

    def view(self, run: int, cache_from: int | None, batch) -> CacheView:
        """What run ``run`` sees: its own pages and states; where it reads the pages of run ``cache_from``, those
        pages (in their order among that run's paged entries) with ``writes`` False."""
        own = iter(zip(self.leaf_tensors[run], self.layout.leaf_group[run]))
        lent = iter(()) if cache_from is None else iter(
            [(pair[0], g) for pair, g in zip(self.leaf_tensors[cache_from], self.layout.leaf_group[cache_from])
             if pair[0] is not None])

        def build(n) -> CacheView:
            if isinstance(n, CompositeNeed):
                return CacheView(children=tuple(build(sub) for sub in n.parts))
            if n is None:
                return CacheView()
            (pages, state), g = next(own)
            if isinstance(n, SharedPagesNeed):
                pages, g = next(lent)
                return CacheView(pages=pages, tables=batch.groups[g], writes=False)
            return CacheView(pages=pages, tables=batch.groups[g] if g is not None else None, state=state)

        return build(self.layout.needs[run])

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for mine in self.leaf_tensors for pair in mine for t in pair
                   if t is not None)
