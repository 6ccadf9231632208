"""Device memory of the cache: page tensors of every group and per-request state.

The reference allocates, per layer, K and V tensors ``[blocks * block_size,
kv_heads, head_dim]`` (inferrs-models/src/kv_cache.rs:249-270).  Here one
tensor per group holds all its caches,

    [caches in group, 2 (keys, values; 1 for a cache of latents), pages, kv_heads, page_size, head_dim]

so that one page of one head is a contiguous ``[page_size, head_dim]`` tile.
Writes are plain stores; a page that is used again needs no clearing because a
request never reads beyond the tokens it has written.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .manager import GroupLayout


@dataclass(frozen=True)
class KVNeed:
    """What a mixer asks of the paged cache for one schedule entry."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    # 2: keys and values each have their pages; 1: one vector per token serves as both (a cache of latents)
    planes: int = 2
    # size of a value head where it differs from a key head's (None: the same; such a group keeps its values in
    # a tensor of their own)
    value_dim: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size that a mixer keeps for one schedule entry."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class CacheStorage:
    def __init__(self, kv_needs: Dict[int, KVNeed], state_needs: Dict[int, StateNeed], page_size: int,
                 n_pages: int, max_requests: int, dtype: torch.dtype, device: torch.device,
                 n_pages_per_group: Optional[Sequence[int]] = None,
                 side_state_needs: Optional[Dict[Tuple[int, Any], StateNeed]] = None):
        """``side_state_needs``: per-request states beside a mixer's own, keyed by (cache id, the description that
        owns the state): the inputs that a short convolution in front of a sub-layer or behind a projection keeps."""
        self.page_size = page_size
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = device
        # caches with equal needs form a group, in order of first appearance
        keys: List[KVNeed] = []
        self.group_of: Dict[int, int] = {}
        self.index_in_group: Dict[int, int] = {}
        members: List[List[int]] = []
        for cid in sorted(kv_needs):
            need = kv_needs[cid]
            if need not in keys:
                keys.append(need)
                members.append([])
            g = keys.index(need)
            self.group_of[cid] = g
            self.index_in_group[cid] = len(members[g])
            members[g].append(cid)
        if not keys:
            # a model whose mixers all keep fixed-size state: one group without caches still counts every request's
            # tokens page by page (positions, the longest context), and holds no memory
            keys.append(KVNeed(n_kv_heads=0, head_dim=0))
            members.append([])
        self.needs = keys
        self.members = members
        if any(k.planes not in (1, 2) for k in keys):
            raise ValueError("a cache has one plane (latents) or two (keys and values)")
        self.layouts = [GroupLayout(name=f"group{g}(heads={k.n_kv_heads},dim={k.head_dim},window={k.window})",
                                    window=k.window) for g, k in enumerate(keys)]
        self.n_pages = list(n_pages_per_group) if n_pages_per_group is not None else [n_pages] * len(keys)
        if any(k.value_dim is not None and k.planes != 2 for k in keys):
            raise ValueError("values of a size of their own need a cache of two planes")
        self.kv: List[torch.Tensor] = []
        # values whose heads have another size than the keys': [caches in group, pages, kv_heads, page_size, value_dim]
        # (the group's tensor in ``kv`` then holds the keys alone)
        self.values: List[Optional[torch.Tensor]] = []
        for g, k in enumerate(keys):
            own_values = k.value_dim is not None and k.value_dim != k.head_dim
            self.kv.append(torch.zeros((len(members[g]), 1 if own_values else k.planes, self.n_pages[g], k.n_kv_heads,
                                        page_size, k.head_dim), dtype=dtype, device=device))
            self.values.append(torch.zeros((len(members[g]), self.n_pages[g], k.n_kv_heads, page_size, k.value_dim),
                                           dtype=dtype, device=device) if own_values else None)
        # one slot more than there are requests: the requests that only pad a replayed step write their state there
        self.states: Dict[int, torch.Tensor] = {
            cid: torch.zeros((max_requests + 1,) + tuple(need.shape), dtype=need.dtype, device=device)
            for cid, need in state_needs.items()}
        self.side_states: Dict[Tuple[int, Any], torch.Tensor] = {
            key: torch.zeros((max_requests + 1,) + tuple(need.shape), dtype=need.dtype, device=device)
            for key, need in (side_state_needs or {}).items()}

    def pages(self, cache_id: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
        """(key pages, value pages, group index) of one cache; pages are [n_pages, kv_heads, page_size, head_dim]
        (value pages end in the group's ``value_dim`` where it has one).
        A cache of one plane gives the same pages twice."""
        g = self.group_of[cache_id]
        t = self.kv[g][self.index_in_group[cache_id]]
        if self.values[g] is not None:
            return t[0], self.values[g][self.index_in_group[cache_id]], g
        return t[0], t[t.shape[0] - 1], g

    def state(self, cache_id: int) -> torch.Tensor:
        return self.states[cache_id]

    def side_state(self, cache_id: int, owner: Any) -> torch.Tensor:
        """The per-request state [slots, ...] that the description ``owner`` keeps under this cache id."""
        return self.side_states[(cache_id, owner)]

    def clear_slot(self, slot: int):
        """A new request takes the slot: its fixed-size states start at zero."""
        for t in list(self.states.values()) + list(self.side_states.values()):
            t[slot].zero_()

    def snapshot_states(self) -> Dict[Any, torch.Tensor]:
        """Copies of all fixed-size states (for a caller that has to run a step more than once)."""
        saved = {cid: t.clone() for cid, t in self.states.items()}
        saved.update({("side",) + key: t.clone() for key, t in self.side_states.items()})
        return saved

    def restore_states(self, saved: Dict[Any, torch.Tensor]):
        for key, t in saved.items():
            if isinstance(key, tuple) and key and key[0] == "side":
                self.side_states[key[1:]].copy_(t)
            else:
                self.states[key].copy_(t)

    def bytes_per_token(self) -> int:
        """Bytes of keys and values that one token adds, over all groups."""
        e = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(self.members[g]) * k.n_kv_heads * (k.head_dim * (k.planes - 1) + (k.value_dim or k.head_dim)) * e
                   for g, k in enumerate(self.needs))

    def total_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * t.element_size() for t in self.values if t is not None) + \
            sum(t.numel() * t.element_size() for t in self.states.values()) + \
            sum(t.numel() * t.element_size() for t in self.side_states.values())
