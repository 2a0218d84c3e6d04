"""Device side of the cache: one key/value pool per group of layers, and per-request state.

Layout of a group's pool: ``[layers of the group, 2 (K, V), pages, kv_heads, page_size, head_dim]``;
for one layer and one of K/V a (page, head) pair is ``page_size * head_dim`` contiguous elements,
which is what the attention kernels stream.  The reference keeps ``[layers, pages, page_size,
kv_heads, head_dim]`` (src/cloud_engine/cache.py:272-274) and sizes the pool from a byte budget
(cache.py:266-271); ``plan_groups`` does the same split here.
"""

from __future__ import annotations

from typing import Any

from ..engine.context import KVLayerView, LayerBinding
from .manager import GroupSpec


def plan_groups(needs: list[Any], element_size: int) -> tuple[list[GroupSpec], dict[int, tuple[int, int]]]:
    """Groups the cache-owning schedule entries by what they need.

    Returns the group list and, per owning entry, (group index, layer index inside the group)."""
    keys: list[tuple[int, int, int]] = []
    members: dict[tuple[int, int, int], list[int]] = {}
    for need in needs:
        if need.pages is None or need.owner != need.entry:
            continue
        key = need.pages.group_key
        if key not in members:
            keys.append(key)
            members[key] = []
        members[key].append(need.entry)
    groups: list[GroupSpec] = []
    place: dict[int, tuple[int, int]] = {}
    for index, key in enumerate(keys):
        window, kv_heads, head_dim = key
        entries = members[key]
        groups.append(
            GroupSpec(
                name=f"window{window}" if window else "full" + (f"-{index}" if index else ""),
                window=window,
                bytes_per_token=2 * kv_heads * head_dim * element_size * len(entries),
            )
        )
        for layer, entry in enumerate(entries):
            place[entry] = (index, layer)
    return groups, place


def pages_from_bytes(groups: list[GroupSpec], page_size: int, budget: int) -> int:
    """Same page count for every group such that all pools together fit ``budget`` bytes
    (one group: cache.py:266-271)."""
    per_page = sum(group.bytes_per_token for group in groups) * page_size
    if per_page == 0:
        return 1
    count = budget // per_page
    if count < 1:
        raise ValueError("kv_cache_bytes too small for even one page")
    return int(count)


class CachePools:
    def __init__(self, needs: list[Any], groups: list[GroupSpec], place: dict[int, tuple[int, int]],
                 pages_per_group: list[int], page_size: int, max_slots: int, dtype: Any,
                 device: Any) -> None:
        import torch

        self.page_size = page_size
        self.pools: list[Any] = []
        shapes: dict[int, tuple[int, int]] = {}
        layers_in: dict[int, int] = {}
        for need in needs:
            if need.entry in place:
                group, layer = place[need.entry]
                shapes[group] = (need.pages.kv_heads, need.pages.head_dim)
                layers_in[group] = max(layers_in.get(group, 0), layer + 1)
        for index, _ in enumerate(groups):
            if index not in shapes:
                self.pools.append(None)
                continue
            kv_heads, head_dim = shapes[index]
            self.pools.append(
                torch.zeros(
                    (layers_in[index], 2, pages_per_group[index], kv_heads, page_size, head_dim),
                    dtype=dtype, device=device,
                )
            )
        self.pages_per_group = list(pages_per_group)
        self.states: dict[int, Any] = {}
        for need in needs:
            if need.state is not None and need.owner == need.entry:
                self.states[need.entry] = torch.zeros(
                    (max_slots, *need.state.shape), dtype=getattr(torch, need.state.dtype),
                    device=device,
                )
        self.bindings: list[LayerBinding] = []
        for need in needs:
            kv = None
            if need.pages is not None:
                group, layer = place[need.owner]
                pool = self.pools[group]
                kv = KVLayerView(group=group, k=pool[layer, 0], v=pool[layer, 1],
                                 num_pages=pages_per_group[group], page_size=page_size)
            self.bindings.append(
                LayerBinding(entry=need.entry, owns_cache=need.owner == need.entry, kv=kv,
                             state=self.states.get(need.owner))
            )

    def zero_slots(self, slots: list[int]) -> None:
        for state in self.states.values():
            for slot in slots:
                state[slot].zero_()

    def bytes_held(self) -> int:
        total = sum(p.numel() * p.element_size() for p in self.pools if p is not None)
        return total + sum(s.numel() * s.element_size() for s in self.states.values())
