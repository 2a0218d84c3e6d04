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


def plan_page_counts(groups: list[GroupSpec], page_size: int, max_requests: int, step_tokens: int = 0,
                     num_pages: int | None = None, kv_cache_bytes: int | None = None) -> list[int]:
    """Pages of every group's pool.  A group that keeps all keys gets ``num_pages`` (or what the
    byte budget allows).  A group that keeps a window of them can never use more than
    ``max_requests`` times the pages of (window + the tokens one request may bring in one step) plus
    one, because pages behind the window go back when a step is committed; it gets no more than
    that, and under a byte budget what it does not need goes to the other groups.  ``step_tokens``
    0 means the bound is not known: every group is sized alike."""
    if not groups:
        return [1]
    caps: list[int | None] = []
    for group in groups:
        if group.window > 0 and step_tokens > 0:
            caps.append(max_requests * (-(-(group.window + step_tokens) // page_size) + 1))
        else:
            caps.append(None)

    def counts(pages: int) -> list[int]:
        return [pages if cap is None else min(pages, cap) for cap in caps]

    if num_pages is not None:
        return counts(int(num_pages))
    if kv_cache_bytes is None:
        raise ValueError("give num_pages or kv_cache_bytes")

    def cost(pages: int) -> int:
        return sum(group.bytes_per_token * page_size * n for group, n in zip(groups, counts(pages)))

    if cost(1) > kv_cache_bytes:
        raise ValueError("kv_cache_bytes too small for even one page")
    low, high = 1, 2
    while cost(high) <= kv_cache_bytes and cost(high) > cost(high // 2):
        low, high = high, high * 2
    if cost(high) <= kv_cache_bytes:      # every group is at its bound: more pages cost nothing more
        return counts(high)
    while high - low > 1:
        middle = (low + high) // 2
        if cost(middle) <= kv_cache_bytes:
            low = middle
        else:
            high = middle
    return counts(low)


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
